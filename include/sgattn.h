/*
 * sgattn.h -- C ABI of libsgattn.so: super-gemma's attention / KV kernels on NVIDIA B200 (sm_100a).
 *
 * The library replaces, for the attention and KV kernels only, the dispatch surface that
 * `sg-model` uses on `sg-gpu` (a Rust API; the reference has no C ABI of its own).  Kernels are
 * addressed exactly as in the reference: by REGISTRY NAME, with a fixed BINDING ORDER, a raw POD
 * PUSH-CONSTANT block and a WORKGROUP GRID; per-step lengths live in the 16-byte STEP BUFFER on
 * the device so that a graph recorded once can be replayed every step.
 * Paths in comments are relative to the reference repository.
 *
 * Threading contract (crates/sg-gpu/src/context.rs:84-85): one submitting thread per context.
 * Every function returns an SGB_* code; sgb_last_error() gives the text of the last failure.
 * There is no CPU fallback: without a usable CUDA device sgb_ctx_create() fails.
 */
#ifndef SGATTN_H
#define SGATTN_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Error codes; the first six mirror `GpuError` (crates/sg-gpu/src/lib.rs:30-44). */
enum {
    SGB_OK = 0,
    SGB_ERR_NO_DEVICE = 1,      /* GpuError::Library / NoDevice */
    SGB_ERR_UNKNOWN_KERNEL = 2, /* GpuError::UnknownKernel */
    SGB_ERR_VALIDATION = 3,     /* GpuError::Validation: binding count, sizes, alignment, page ids */
    SGB_ERR_CUDA = 4,           /* GpuError::Vk / Pipeline: a CUDA runtime or driver call failed */
    SGB_ERR_TIMEOUT = 5,        /* a bounded wait ran out (host sync, or a device-side wait) */
    SGB_ERR_BOUNDS = 6,         /* a kernel recorded an out-of-range index in the status word */
    SGB_ERR_STATE = 7           /* call not legal now (e.g. graph_end without graph_begin) */
};

typedef struct sgb_ctx sgb_ctx;
typedef struct sgb_buffer sgb_buffer;
typedef struct sgb_kernel sgb_kernel;
typedef struct sgb_graph sgb_graph;
typedef struct sgb_timer sgb_timer;

/* Library version and the text of the calling thread's last error. */
const char *sgb_version(void);
const char *sgb_last_error(void);

/* ---- context: GpuContext::new (crates/sg-gpu/src/context.rs:103) ------------------------------ */
/* One CUDA device, one stream.  sgb_ctx_create makes its own stream; `stream` (a cudaStream_t, NULL =
 * the legacy default stream) lets a host
 * that already owns a stream (e.g. a PyTorch process doing NCCL on it) order its work with ours. */
int sgb_ctx_create(int device, sgb_ctx **out);
int sgb_ctx_create_on_stream(int device, void *stream, sgb_ctx **out);
void sgb_ctx_destroy(sgb_ctx *ctx);
int sgb_ctx_device(const sgb_ctx *ctx);
void *sgb_ctx_stream(const sgb_ctx *ctx);
int sgb_ctx_sm_count(const sgb_ctx *ctx);

/* Completion: submit_and_wait (crates/sg-gpu/src/graph.rs:645-667), but with a FINITE wait.
 * Also reads and clears the device status word, so device-side SGB_ERR_TIMEOUT / SGB_ERR_BOUNDS
 * surface here.  timeout_ms = 0 means 30 s. */
int sgb_sync(sgb_ctx *ctx, uint32_t timeout_ms);

/* ---- buffers: Buffer<T> (crates/sg-gpu/src/buffer.rs:80,112-162,257-278) ---------------------- */
/* Device memory; create() zero-fills as new_buffer does.  The reference maps unified memory into
 * the host; here upload/download are explicit copies ordered on the context's stream.  The
 * *_async forms return at once (give them pinned host memory); the plain forms wait. */
int sgb_buffer_create(sgb_ctx *ctx, size_t bytes, sgb_buffer **out);
int sgb_buffer_adopt(sgb_ctx *ctx, void *device_ptr, size_t bytes, sgb_buffer **out); /* not owned */
int sgb_buffer_slice(sgb_buffer *parent, size_t offset, size_t bytes, sgb_buffer **out); /* Buffer::slice */
void sgb_buffer_retain(sgb_buffer *buf);
void sgb_buffer_release(sgb_buffer *buf);
void *sgb_buffer_device_ptr(const sgb_buffer *buf);
size_t sgb_buffer_bytes(const sgb_buffer *buf);
int sgb_buffer_upload(sgb_buffer *buf, size_t offset, const void *host, size_t bytes);
int sgb_buffer_download(sgb_buffer *buf, size_t offset, void *host, size_t bytes);
int sgb_buffer_upload_async(sgb_buffer *buf, size_t offset, const void *host, size_t bytes);
int sgb_buffer_download_async(sgb_buffer *buf, size_t offset, void *host, size_t bytes);
int sgb_buffer_fill_zero(sgb_buffer *buf);
int sgb_host_alloc(size_t bytes, void **out); /* pinned host memory for the async copies */
void sgb_host_free(void *p);

/* StepState::write_to (crates/sg-gpu/src/graph.rs:29-61): u32[4] = pos, kv_len_sliding,
 * kv_len_global, q0.  Ordered on the stream, so it may be called between graph launches. */
int sgb_step_write(sgb_buffer *step, uint32_t pos, uint32_t kv_len_sliding, uint32_t kv_len_global, uint32_t q0);

/* ---- kernel registry: KERNELS / kernel_blob / load_kernel (crates/sg-gpu/src/kernel.rs:18-41,79) */
typedef struct {
    const char *name;
    uint32_t workgroup[3]; /* threads per workgroup of the REFERENCE variant (informational) */
    uint32_t bindings;     /* number of storage-buffer bindings, indices 0..bindings-1 */
    uint32_t push_bytes;   /* size of the push-constant block, 0 = none */
    const char *signature; /* binding order, push layout and grid meaning, as text */
} sgb_kernel_info;

int sgb_kernel_count(void);
int sgb_kernel_info_at(int index, sgb_kernel_info *out);
int sgb_kernel_get(sgb_ctx *ctx, const char *name, sgb_kernel **out); /* SGB_ERR_UNKNOWN_KERNEL on a miss */
int sgb_kernel_describe(const sgb_kernel *k, sgb_kernel_info *out);

/* ---- dispatch: GraphRecorder::dispatch (crates/sg-gpu/src/graph.rs:203-211) and -------------- */
/* dispatch_blocking (crates/sg-gpu/src/exec.rs:12-23).  Bindings are (index, buffer view); the  */
/* push block is raw bytes of exactly push_bytes; groups keeps the reference's grid meaning per  */
/* kernel (see `signature`).  Work is ordered on the stream, which gives the compute->compute    */
/* barrier the reference recorder inserts before every dispatch (graph.rs:269-273).              */
/* One kernel family allocates behind the caller's back: attn_prefill_flash_f16_d128 and         */
/* attn_prefill_paged_q8kv_flash_d128 cut long key ranges into pieces to fill the last wave of   */
/* CTAs, and keep the pieces' partial results (rows x pieces x 130 floats; 136 MB for a          */
/* 4096-token chunk of 32 heads in 2 pieces) in a scratch block that the first dispatch needing  */
/* it cudaMallocs per (device, stream) and the library keeps until the process exits.  A         */
/* dispatch made while a graph is being recorded never allocates: with no block from an earlier  */
/* dispatch it runs the same kernel without cutting (same results within rounding, a few per     */
/* cent slower), so make one un-recorded dispatch of the shape first if the recorded one should  */
/* cut.  No other kernel of the registry allocates.                                              */
typedef struct {
    uint32_t index;
    sgb_buffer *buffer;
} sgb_binding;

int sgb_dispatch(sgb_ctx *ctx, const sgb_kernel *k, const sgb_binding *bindings, uint32_t n_bindings, const void *push,
                 size_t push_bytes, const uint32_t groups[3]);
int sgb_dispatch_blocking(sgb_ctx *ctx, const sgb_kernel *k, const sgb_binding *bindings, uint32_t n_bindings,
                          const void *push, size_t push_bytes, const uint32_t groups[3]);
/* How many of this library's kernels have been launched through ctx (graph replays included). */
uint64_t sgb_launch_count(const sgb_ctx *ctx);
/* A split count for attn_decode_paged_q8kv_d128 / attn_verify_paged_q8kv_d128 that fills every SM of this
 * device evenly (the reference keeps n_splits as a policy constant, SPLITS_GLOBAL = 32, crates/sg-model/src/graph.rs:37;
 * any value stays valid, this one measured 5-12 % faster than 64 on 148 SMs).  At least 512 tokens per split.
 * (sgb_decode_paged_q8kv_d128_noalloc caps m_q * q_heads * n_splits at 2048: 64 splits for 32 q heads.) */
uint32_t sgb_decode_paged_splits_hint(const sgb_ctx *ctx, uint32_t n_kv_heads, uint32_t kv_len);

/* ---- record once, replay: record_graph / submit_blocking (crates/sg-gpu/src/graph.rs:523-528, */
/* 640-642).  Between begin and end every sgb_dispatch / sgb_step_write-free call is captured    */
/* into a CUDA graph instead of running; the graph keeps its buffers alive.                      */
int sgb_graph_begin(sgb_ctx *ctx);
int sgb_graph_end(sgb_ctx *ctx, sgb_graph **out);
int sgb_graph_launch(sgb_ctx *ctx, sgb_graph *g); /* asynchronous; follow with sgb_sync */
void sgb_graph_destroy(sgb_graph *g);

/* ---- timers: GpuTimer (crates/sg-gpu/src/graph.rs:334-381,404-473) ---------------------------- */
int sgb_timer_create(sgb_ctx *ctx, uint32_t n_stamps, sgb_timer **out);
int sgb_timer_stamp(sgb_ctx *ctx, sgb_timer *t, uint32_t index); /* also legal while recording */
int sgb_timer_read_ns(sgb_timer *t, uint64_t *out_ns, uint32_t n); /* ns since stamp 0; syncs the events */
void sgb_timer_destroy(sgb_timer *t);

/* ---- cache2 page tables: the radix trie of docs/plans/04-kv-cache.md:40-51 and the page-size ---- */
/* constants of crates/sg-cache/src/lib.rs:9-13 (the reference has the design only, no code).     */
/* Host-side and device-free: a trie keyed by whole pages of token ids over a pool of `pool_pages` */
/* physical KV pages of `page_tokens` tokens (a power of two in 16..512).  It produces the        */
/* page_table the paged kernels read; the caller uploads it with sgb_buffer_upload.  Single        */
/* writer, like the reference's design: calls on one handle must not overlap.                      */
typedef struct sgb_cache2 sgb_cache2;
typedef struct sgb_cache2_stats_t {
    uint32_t page_tokens, pool_pages, free_pages, reclaimable_pages, live_sequences, reserved;
    uint64_t hits, misses, evictions;
} sgb_cache2_stats_t;
int sgb_cache2_create(uint32_t page_tokens, uint32_t pool_pages, sgb_cache2 **out);
void sgb_cache2_destroy(sgb_cache2 *c);
/* Longest cached page-aligned prefix of `tokens`, in tokens (04-kv-cache.md:46). No state change. */
int sgb_cache2_lookup(sgb_cache2 *c, const int32_t *tokens, uint64_t n_tokens, uint64_t *matched_tokens);
/* Start a sequence that knows `n_tokens` token ids and may grow to `capacity_tokens`: the pages of
 * its longest cached prefix are shared (their K/V is already in the pool: the caller appends from
 * token `*reused_tokens` on), private pages are taken for the rest -- from the free list, else by
 * reclaiming least-recently-used cached pages that no live sequence holds.  Writes the logical ->
 * physical page list to table[0..*n_pages) and a handle to *seq.  SGB_ERR_STATE and no change when
 * the pool cannot supply the pages; SGB_ERR_VALIDATION when table_capacity is too small. */
int sgb_cache2_acquire(sgb_cache2 *c, const int32_t *tokens, uint64_t n_tokens, uint64_t capacity_tokens, uint32_t *table,
                       uint32_t table_capacity, uint32_t *n_pages, uint64_t *reused_tokens, uint64_t *seq);
/* Insert on commit (04-kv-cache.md:47-48): the sequence's private pages that tokens[0..n_tokens)
 * fill completely become shareable trie nodes (the sequence keeps holding them).  Call it once their
 * K/V is in the pool.  The physical page list of the sequence does not change. */
int sgb_cache2_commit(sgb_cache2 *c, uint64_t seq, const int32_t *tokens, uint64_t n_tokens);
/* End a sequence: private pages go back to the free list, shared ones stay cached until reclaimed. */
int sgb_cache2_release(sgb_cache2 *c, uint64_t seq);
int sgb_cache2_stats(const sgb_cache2 *c, sgb_cache2_stats_t *out);

/* ---- allocation-free decode (no counterpart in the reference) ---------------------------------- */
/* For hosts that cannot allocate device memory when they need attention -- a serving process that
 * has given all of HBM to its KV pool, or a caller inside a phase where cudaMalloc is off limits.
 * Runs the whole decode step of attn_decode_paged_q8kv_d128 + attn_reduce_f32_d128 (same layouts,
 * same arithmetic) on `stream` without cudaMalloc, cudaFree or any allocating library call: the
 * split-K partials and the step words live in a static device array inside the library (about
 * 1.04 MB, held by every GPU that loads the library until the process exits).
 *   q f16 [m_q x n_kv_heads*2 x 128]; K/V pools as in the kernel signature (pool_rows rows each);
 *   page_table u32[table_len]; out f32 [m_q x n_kv_heads*2 x 128]; status: NULL or 4 x u32 of device
 *   memory that receives a device-side error report (first word non-zero = SGB_ERR_* code).
 * Limit: m_q * n_kv_heads*2 * n_splits <= 2048 partial rows (32 q heads x 64 splits); larger
 * requests are rejected with SGB_ERR_VALIDATION.  All arguments are device pointers owned by the
 * caller; the call is asynchronous on `stream` (NULL = the legacy default stream).
 * The first call on each device resolves the static array's address and sets a kernel attribute:
 * make that first call outside any stream capture.  That first call is also where the CUDA runtime
 * loads the library's device code on that device (module loading is lazy), and loading is when the
 * driver sets the static array's 1.04 MB aside: a host that is about to commit every remaining byte
 * of HBM must make one call per device BEFORE it does so; later calls leave free device memory
 * unchanged.  The set-up is serialised by a lock, so first calls may come from several threads.
 * kv_len counts the m_q query tokens themselves (append, then attend): kv_len < m_q is rejected.
 * Every call shares the one array and leaves its
 * last partials there (each call overwrites all rows it reads, nothing needs zeroing); two calls
 * that overlap on the GPU -- different streams, or different threads -- race on it. */
int sgb_decode_paged_q8kv_d128_noalloc(int device, void *stream, const void *q, const void *k_quants, const void *k_scales,
                                       const void *v_quants, const void *v_scales, const uint32_t *page_table,
                                       uint32_t table_len, uint64_t pool_rows, float *out, uint32_t *status,
                                       uint32_t n_kv_heads, uint32_t m_q, uint32_t kv_len, uint32_t n_splits, uint32_t page,
                                       float scale);

#ifdef __cplusplus
}
#endif
#endif /* SGATTN_H */
