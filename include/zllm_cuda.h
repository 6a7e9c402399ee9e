/* zllm_cuda: a CUDA (sm_100a) host for zllm's backend command stream.
 *
 * The B200 counterpart of the reference's native D3D12 host: a thin C
 * interface (compare src/agility/agility.h:21-130) that the Zig side binds
 * through translate-c, with the same conventions: opaque handles, int32
 * results where negative means failure, a last-error string per context,
 * serialized access per context, explicit timeouts on every wait.
 *
 * Two levels are exported:
 *   1. zcu_execute: interprets one batch of the command stream exactly as
 *      src/gpu/cmd.zig:21-59 encodes it and src/agility/host.zig:311-607
 *      executes it (writes first, ops in order, blocking submit, one
 *      completion per read and per submit).
 *   2. zcu_launch and the buffer calls: one kernel dispatch with explicit
 *      bindings, for callers that hold device pointers already (benchmarks,
 *      the kernel check, the tuning sweep).
 *
 * Kernel identities are the values of the reference's `Kernel` enum
 * (src/kernels/kernels.zig:24-101); parameter blocks are its `params.*`
 * extern structs (src/kernels/kernels.zig:432-650), bit for bit; bindings
 * follow each kernel's declared binding order.
 */
#ifndef ZLLM_CUDA_H
#define ZLLM_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ZCU_ABI_VERSION 1u

typedef struct zcu_context zcu_context;
typedef int32_t zcu_result;

/* Results. Negative values are failures and map onto the Zig host's error
 * set (src/agility/host.zig:38, src/gpu/cmd.zig:222). */
enum {
    ZCU_OK = 0,
    ZCU_E_GPU = -1,                /* error.GpuError */
    ZCU_E_DEVICE_LOST = -2,        /* error.DeviceLost */
    ZCU_E_BAD_COMMAND = -3,        /* error.BadCommand */
    ZCU_E_BAD_ID = -4,             /* error.BadId */
    ZCU_E_NO_TIMESTAMPS = -5,      /* error.NoTimestamps */
    ZCU_E_UNSUPPORTED_KERNEL = -6, /* error.UnsupportedKernel */
    ZCU_E_UNSUPPORTED_PREFILL = -7,/* error.UnsupportedPrefill */
    ZCU_E_TRUNCATED = -8,          /* cmd.DecodeError.Truncated */
    ZCU_E_BAD_LENGTH = -9,         /* cmd.DecodeError.BadLength */
    ZCU_E_OUT_OF_MEMORY = -10,     /* error.OutOfMemory */
    ZCU_E_TIMEOUT = -11,           /* a wait ran out (reported as GpuError upstream) */
    ZCU_E_INVALID = -12            /* a bad argument to this interface */
};

/* Notes on identities whose dispatch differs in shape from the reference's (parameter blocks and bindings are the
 * reference's in every case):
 *   ZCU_K_SAMPLE       the dispatch of phase 0 (prep) makes the whole draw in one cooperative launch; phases 1-10 are
 *                      accepted and launch nothing; phase 11 (unbump) undoes the count (src/kernels/sample.wgsl)
 *   ZCU_K_REPAD, ZCU_K_REPACK_Q3_K   file blocks -> kernels.blockStride layouts; ZCU_K_MATVEC_Q3_K/Q5_K/Q6_K and the
 *                      matching embeds read those (Embed.stride != 0: file layout)
 * Kernel identities: @intFromEnum(kernels.Kernel), src/kernels/kernels.zig:24-101.
 * Only the identities of the decode/prefill path are implemented; the rest
 * report "missing" (an empty artifact) exactly as a backend that lacks a
 * kernel does (src/kernels/kernels.zig:752-755). */
enum {
    ZCU_K_RMSNORM = 0,
    ZCU_K_MATMUL_BF16 = 1,
    ZCU_K_MATMUL_F16 = 2,
    ZCU_K_MATMUL_REDUCE = 3,
    ZCU_K_MATVEC_BF16 = 4,
    ZCU_K_MATVEC_F16 = 5,
    ZCU_K_SILU_MUL = 6,
    ZCU_K_EMBED_BF16 = 7,
    ZCU_K_EMBED_F16 = 8,
    ZCU_K_ROPE_APPEND = 9,
    ZCU_K_ATTN_SPLIT = 10,
    ZCU_K_ATTN_SPLIT_WIDE = 11,
    ZCU_K_ATTN_COMBINE = 13,
    ZCU_K_DELTA_PREP = 18,
    ZCU_K_DELTA_RULE = 19,
    ZCU_K_GATED_NORM = 20,
    ZCU_K_MARK_TOKENS = 21,
    ZCU_K_SAMPLE = 22,
    ZCU_K_DRAFT = 23,
    ZCU_K_REPAD = 36,
    ZCU_K_REPACK_Q3_K = 37,
    ZCU_K_REPACK_Q8_0 = 38,
    ZCU_K_QUANTIZE_Q8 = 39,
    ZCU_K_MATVEC_Q8_0 = 40,
    ZCU_K_MATVEC_Q3_K = 41,
    ZCU_K_MATVEC_Q4_K = 42,
    ZCU_K_MATVEC_Q5_K = 43,
    ZCU_K_MATVEC_Q6_K = 44,
    ZCU_K_MATMUL_Q8_0 = 45,
    ZCU_K_MATMUL_Q8_0_FLOAT = 46,
    ZCU_K_MATMUL_Q4_K = 48,
    ZCU_K_EMBED_Q8_0 = 51,
    ZCU_K_EMBED_Q3_K = 52,
    ZCU_K_EMBED_Q4_K = 53,
    ZCU_K_EMBED_Q5_K = 54,
    ZCU_K_EMBED_Q6_K = 55,
    ZCU_K_EMBED_IQ4_XS = 56,
    ZCU_K_COUNT = 57,
    /* identities of this backend only (above the reference's enum) */
    ZCU_K_EXT_PEER_WAIT = 64,  /* waits for one tensor-parallel exchange; parameter block = zcu_peer_ext; binding: the vector */
    ZCU_K_EXT_PEER_NEXT = 65   /* ends a run of a launch list that uses exchanges; parameter block = zcu_peer_ext, its slots unused */
};

/* Variant ids of a matvec pipeline (create_kernel's `variant`). 0 is the
 * default. The reference packs (wg/32) | lanes<<8 | rows<<16 | act_div<<24
 * (src/kernels/kernels.zig:330-333); this backend reads the same word as
 * weight tiles in flight per warp (byte 0: 2..6; 0 = as deep as fits),
 * the CTA shape (byte 1: low nibble 0 = CTAs of 16 warps, 1 = of 8 warps, two
 * per SM; bit 4 = a CTA on every SM instead of the count that divides the row
 * tiles evenly), and kernel family (byte 2: 1 = scalar f32 FMA,
 * 2 = integer tensor-core fragments, 3 = matvec_q4_k for up to 64 tokens in
 * one pass over the weights: tcgen05 with accumulators in tensor memory, the
 * tokens as two f16 terms; bytes 0 and 1 zero). The whole word 0 on
 * matvec_q4_k is ZCU_VARIANT(3, 0x10, ZCU_FAMILY_MMA), what a load-time
 * sweep ends up choosing for the shapes of a decode step. Reserved
 * prefill rungs keep the reference's ids (src/kernels/kernels.zig:798-822). */
#define ZCU_VARIANT(tiles, splitk, family) ((uint32_t)(tiles) | ((uint32_t)(splitk) << 8) | ((uint32_t)(family) << 16))
#define ZCU_FAMILY_SCALAR 1u
#define ZCU_FAMILY_MMA 2u
#define ZCU_FAMILY_TCGEN05 3u
#define ZCU_VARIANT_PREFILL_BF16_TC 0xfffc0000u
/* delta_rule in its chunked form (64-token chunks, the remainder by the recurrent kernel). No reference
 * counterpart: the reference runs every token serially. DeltaRule._pad must hold the step's token count. */
#define ZCU_VARIANT_DELTA_CHUNK64 0xfffd0000u
/* the same chunked form in f32 on the CUDA cores (the default runs its contractions on the tensor cores) */
#define ZCU_VARIANT_DELTA_CHUNK64_F32 0xfffd0001u

typedef struct zcu_options {
    uint32_t abi_version;  /* ZCU_ABI_VERSION */
    uint32_t device_index; /* CUDA ordinal (the reference's adapter index, src/gpu/host.zig:52-57) */
    uint32_t dry_run;      /* 1: no device; buffers live in host memory, dispatches are validated
                              and counted but never executed (command-stream tests on a CPU box) */
    uint32_t reserved;
    void *stream;          /* a cudaStream_t to launch on, or NULL for a stream the context owns */
} zcu_options;

typedef struct zcu_caps {
    uint32_t abi_version;
    uint32_t sm_major;
    uint32_t sm_minor;
    uint32_t sm_count;
    uint32_t max_shared_per_block;
    uint32_t l2_bytes;
    uint64_t total_bytes;
    uint64_t free_bytes;
    uint32_t max_binding_lo; /* Device.limits(): max_binding (u64 split), offset_align */
    uint32_t max_binding_hi;
    uint32_t offset_align;
    uint32_t dry_run;
    char device_name[128];
} zcu_caps;

/* cmd.Completion (src/gpu/cmd.zig:89-95). */
typedef struct zcu_completion {
    uint32_t token;
    uint32_t status; /* 0 ok, 1 failed */
} zcu_completion;

/* One bound range: a device pointer (buffer base + offset) and its size. */
typedef struct zcu_binding {
    void *ptr;
    uint64_t size;
} zcu_binding;

/* gpu.Timings rows (src/gpu/timings.zig:6-27): totals per (kernel, grid). */
typedef struct zcu_timing {
    uint32_t kernel;
    uint32_t variant;
    uint32_t grid[3];
    uint32_t count;
    double total_us;
} zcu_timing;

/* ---- context (replaces Device.open/deinit/limits/memoryBudget/adapter/errorMessage/forceLoss,
 *      src/gpu/host.zig:48-136; vel_create/vel_get_caps/vel_last_error/vel_remove_device/vel_destroy,
 *      src/agility/agility.h:72-73,107-111,130) */
zcu_result zcu_create(const zcu_options *options, zcu_context **out_context);
zcu_result zcu_destroy(zcu_context *context, uint32_t timeout_ms);
zcu_result zcu_get_caps(zcu_context *context, zcu_caps *out_caps);
/* Copies the last error message (NUL-terminated); returns its length. */
size_t zcu_last_error(zcu_context *context, char *out, size_t capacity);
/* Marks the device lost on the host: every later call fails with
 * ZCU_E_DEVICE_LOST. No GPU fault is raised (lost-device tests,
 * src/gpu/host.zig:130-135). */
zcu_result zcu_force_loss(zcu_context *context);
/* Device.memoryBudget (src/gpu/host.zig:76-84): bytes a model may take. */
zcu_result zcu_memory_budget(zcu_context *context, uint64_t *out_bytes);
/* A string that changes whenever any kernel of this backend changes: the
 * plan-cache key input `backendSource` (src/plan/cache.zig:56-85). */
const char *zcu_backend_source(void);
/* The artifact `kernels.artifact(.cuda, k, variant)` passes to create_kernel
 * (src/kernels/kernels.zig:904-922): a short name, or an empty string (length
 * 0) for an identity or variant this backend lacks. Returns its length. */
size_t zcu_artifact(uint32_t kernel, uint32_t variant, char *out, size_t capacity);
/* Device.supportsPrefill(rung) (src/gpu/host.zig:120-128): 1 or 0. */
int32_t zcu_supports_prefill(zcu_context *context, uint32_t rung_variant);

/* Flags of the matvec_* parameter block beyond the reference's (NORM = 1, ACCUMULATE = 2, SILU_PAIR = 4), both for
 * the tensor-core family of matvec_q4_k / matvec_q8_0:
 *   8  the outputs are a Q|K|V row: rope_append's work happens in the multiply's epilogue. Parameter block: MatvecBf16
 *      followed by RopeAppend; bindings 4.. = rope_append's table, kc, vc, step[, positions] (binding 3 = norm weights).
 *   16 the input is the attention output and attn_combine has not run: the multiply's first CTAs merge attn_split's
 *      partials and push the heads as the exchange the multiply itself waits for. Parameter block: MatvecBf16 followed
 *      by Attention, then a zcu_peer_ext with a wait_slot; bindings 4.. = attn_combine's qg, part, out, step[, positions]
 *      (`out` = where attn_combine would write, inside the local arena). */
#define ZCU_MV_ROPE_APPEND 8u
#define ZCU_MV_ATTN_COMBINE 16u

/* The RoPE table rope_append reads: f32 (cos, sin) at (pos * n_rot/2 + i) * 2 with
 * theta = pos * base^(-2i/n_rot) / factors[i], all in f32 (kernels.ropeTableScaled,
 * src/kernels/kernels.zig:730-744; formula of src/ref/ops.zig:95-99). `factors` may be NULL.
 * Host code only: no device is touched. */
zcu_result zcu_rope_table(float *out, uint32_t positions, uint32_t n_rot, float base, const float *factors);

/* ---- command stream (replaces Host.execute/setFile/startProfile/stopProfile/timings,
 *      src/gpu/host.zig:138-191; semantics of src/agility/host.zig:293-607) */
/* `words` is one batch (src/gpu/cmd.zig:9-13). Blocks at every submit until the
 * device has finished it (or timeout_ms passes). Appends completions to `out`
 * (capacity `cap`), the count to `n_out`. The caller owns `words`, every
 * write source and every read destination until this returns. */
zcu_result zcu_execute(zcu_context *context, const uint32_t *words, size_t n_words, zcu_completion *out,
                       size_t cap, size_t *n_out, uint32_t timeout_ms);
/* The mapped model file that write_file commands copy from. */
zcu_result zcu_set_file(zcu_context *context, const void *mapped, uint64_t length, const char *path);
zcu_result zcu_start_profile(zcu_context *context);
zcu_result zcu_stop_profile(zcu_context *context);
/* Copies up to `cap` timing rows; `n_out` gets the number available. */
zcu_result zcu_read_timings(zcu_context *context, zcu_timing *out, size_t cap, size_t *n_out);

/* ---- direct level (replaces vel_create_resource / vel_dispatch / vel_readback / vel_wait_compute,
 *      src/agility/agility.h:103-123, for callers that skip the stream) */
zcu_result zcu_alloc(zcu_context *context, uint64_t bytes, void **out_ptr);
zcu_result zcu_free(zcu_context *context, void *ptr);
zcu_result zcu_upload(zcu_context *context, void *dst, const void *src, uint64_t bytes);   /* async on the stream */
zcu_result zcu_download(zcu_context *context, void *dst, const void *src, uint64_t bytes); /* blocks */
zcu_result zcu_memset(zcu_context *context, void *dst, int value, uint64_t bytes);
/* One dispatch of `kernel` in `variant`. `params` is the kernel's binding-0
 * block (host memory, `params_bytes` long); `bindings[i]` is binding i+1.
 * `grid` is the reference's workgroup grid for the dispatch
 * (kernels.Grid, src/kernels/kernels.zig:990-1043): this backend takes the
 * token count and key blocks from it and sizes its own CUDA grid. */
zcu_result zcu_launch(zcu_context *context, uint32_t kernel, uint32_t variant, const void *params,
                      uint32_t params_bytes, const zcu_binding *bindings, uint32_t n_bindings,
                      const uint32_t grid[3]);
zcu_result zcu_sync(zcu_context *context, uint32_t timeout_ms);
/* Number of kernel launches this context has issued (dry runs count too). */
uint64_t zcu_launch_count(zcu_context *context);

/* Decode attention (attn_split + attn_combine in one call) that allocates nothing. It has no counterpart
 * in the reference. It exists for callers that cannot call cudaMalloc: hosts that were handed fixed input
 * and output buffers and no memory budget of their own, or code on a path where an allocation's implicit
 * device synchronisation is not acceptable. The per-block partials, which attn_split normally writes to a
 * caller-allocated buffer, go to a fixed 4 MiB array inside the library instead (held by every GPU that
 * loads the library until the process exits).
 *   params:   the reference's Attention block (48 bytes); its max_blocks field is ignored
 *   bindings: qg, kc, vc, out, step [, per-row positions when params._pad[0] != 0]
 *   max_keys: the largest position + 1 any row attends to; rows: tokens (or sequences) in the step
 * Limit: rows * heads * ceil(max_keys / 64) * (head_dim + 2) <= 1 Mi floats, else ZCU_E_INVALID with a
 * message (e.g. 32 heads of 128 at up to 16 000 positions for one row). The first call on a device looks
 * the array's address up; make that call before any stream capture. Every call uses the same array, so two
 * calls that overlap on the GPU (different streams or contexts of one process) race; calls on one stream
 * do not. Nothing in the array needs clearing between calls: each call writes every slot it later reads. */
zcu_result zcu_attention_decode_static(zcu_context *context, const void *params, uint32_t params_bytes,
                                       const zcu_binding *bindings, uint32_t n_bindings, uint32_t max_keys,
                                       uint32_t rows);

/* Replays of a fixed launch list: everything issued between begin and end
 * is captured into one CUDA graph instead of running. Step-dependent kernels
 * read their Step block (src/kernels/kernels.zig:436) from device memory, so
 * one graph serves every step whose grids do not change. */
zcu_result zcu_capture_begin(zcu_context *context);
zcu_result zcu_capture_end(zcu_context *context, uint32_t *out_graph);
zcu_result zcu_graph_launch(zcu_context *context, uint32_t graph);
zcu_result zcu_graph_destroy(zcu_context *context, uint32_t graph);

/* Tensor-parallel exchange over peer memory, one process per GPU (no collective library, no multicast, no
 * fences). Every rank allocates one arena (zcu_alloc), exports it (zcu_ipc_export: a 64-byte handle for the other
 * processes), opens its peers' (zcu_ipc_open) and calls zcu_peer_config with all bases as mapped locally. The
 * first `exchange_offset` bytes hold the vectors that every rank reads whole; the 2 * exchange_offset bytes after
 * them are their exchange slots: 8 bytes {value, tag} per float. A dispatch takes part by appending a zcu_peer_ext
 * to its parameter block: matvec_q4_k/q8_0 (tensor-core family) and attn_combine with `push_slot` also store each
 * output, tagged, into the slot of every rank; matvec_* with `wait_slot` read their activations from the slots
 * and wait, element by element, for the tag of the exchange; ZCU_K_EXT_PEER_WAIT (binding: the vector) waits the
 * same way and fills in the plain floats, for a host about to read them. Tags derive from the slot and from an
 * epoch, a local word that counts the runs of the launch list: a list that uses exchanges and runs more than once
 * (a replayed step) ends with ZCU_K_EXT_PEER_NEXT, which moves the epoch on; within a run a slot is written by at
 * most one dispatch (however many launches that dispatch takes). The reference has no multi-GPU path;
 * this is the row/head sharding its kernels allow (every output row, head and state column is computed by one
 * rank with unchanged arithmetic, so results are bitwise those of one GPU). A wait gives up after 2 s (or the limit
 * set by zcu_peer_wait_limit) with ZCU_E_GPU at the next sync; every later wait of the context then gives up at once
 * until zcu_peer_config is called again. zcu_peer_config zeroes this rank's exchange slots: every rank must have
 * returned from it (a barrier of the caller's) before any rank launches a kernel that pushes; and it must not be
 * called again while graphs captured under the old configuration are still replayed. */
#define ZCU_PEER_MAGIC 0x52454550u
#define ZCU_PEER_NONE 0xffffffffu
typedef struct zcu_peer_ext {
    uint32_t magic;     /* ZCU_PEER_MAGIC */
    uint32_t wait_slot; /* or ZCU_PEER_NONE */
    uint32_t push_slot; /* or ZCU_PEER_NONE */
    uint32_t reserved;
} zcu_peer_ext;
zcu_result zcu_ipc_export(zcu_context *context, void *ptr, void *out_handle64);
zcu_result zcu_ipc_open(zcu_context *context, const void *handle64, void **out_ptr);
zcu_result zcu_peer_config(zcu_context *context, uint32_t rank, uint32_t world, const uint64_t *bases, uint64_t arena_bytes,
                           uint64_t exchange_offset, uint32_t slots);
/* How long a kernel waits for a slice of an exchange before it gives up (launches from now on; 0 = 2000 ms). */
zcu_result zcu_peer_wait_limit(zcu_context *context, uint32_t milliseconds);

#ifdef __cplusplus
}
#endif
#endif
