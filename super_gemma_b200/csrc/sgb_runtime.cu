// Host runtime behind the C ABI of include/sgattn.h: context, buffers, kernel lookup, dispatch,
// record/replay and timers.  It mirrors the slice of sg-gpu that the attention path uses
// (crates/sg-gpu/src/{context,buffer,kernel,graph,exec}.rs); the Vulkan objects become a CUDA
// stream, device allocations, CUDA graphs and events.
#include <cuda.h>
#include <cuda_runtime.h>

#include <atomic>
#include <chrono>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

#include "../../include/sgattn.h"
#include "sgb_kernels.h"

namespace sgb {

static thread_local std::string g_last_error;

static int set_error(int code, const std::string& msg)
{
    g_last_error = msg;
    return code;
}

int set_last_error(int code, const std::string& msg) { return set_error(code, msg); }

bool pdl_enabled()
{
    static const bool on = [] {
        const char* e = getenv("SGB_PDL");
        return !(e && e[0] == '0');
    }();
    return on;
}

int fail_validation(const LaunchArgs& a, const std::string& msg)
{
    if (a.err) *a.err = msg;
    return SGB_ERR_VALIDATION;
}

int check_cuda(const LaunchArgs& a, cudaError_t e, const char* what)
{
    if (e == cudaSuccess) return SGB_OK;
    if (a.err) *a.err = std::string(what) + ": " + cudaGetErrorString(e);
    return SGB_ERR_CUDA;
}

int need_bytes(const LaunchArgs& a, int binding, size_t bytes, const char* what)
{
    if (a.b[binding].bytes >= bytes) return SGB_OK;
    char buf[256];
    snprintf(buf, sizeof buf, "binding %d (%s) holds %zu bytes, the kernel needs %zu", binding, what, a.b[binding].bytes,
             bytes);
    return fail_validation(a, buf);
}

// cuTensorMapEncodeTiled, looked up through the runtime so the library has no link-time
// dependency on libcuda (it must load, and export its symbols, on a machine without a driver).
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn()
{
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

int encode_tensor_map(const LaunchArgs& a, void* out_map, int elem_kind, int rank, void* base, const uint64_t* dims,
                      const uint64_t* strides_bytes, const uint32_t* box, int swizzle)
{
    EncodeTiledFn fn = encode_fn();
    if (!fn) {
        if (a.err) *a.err = "cuTensorMapEncodeTiled is not available from this driver";
        return SGB_ERR_CUDA;
    }
    cuuint64_t gd[5], gs[5];
    cuuint32_t bx[5], es[5];
    for (int i = 0; i < rank; i++) {
        gd[i] = dims[i];
        bx[i] = box[i];
        es[i] = 1;
        if (i + 1 < rank) gs[i] = strides_bytes[i];
    }
    const CUresult r = fn(reinterpret_cast<CUtensorMap*>(out_map),
                          elem_kind == 0 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, (cuuint32_t)rank,
                          base, gd, gs, bx, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          swizzle == 3 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        char buf[160];
        snprintf(buf, sizeof buf, "cuTensorMapEncodeTiled failed with CUresult %d (rank %d, base %p)", (int)r, rank, base);
        if (a.err) *a.err = buf;
        return SGB_ERR_VALIDATION;
    }
    return SGB_OK;
}

}  // namespace sgb

using namespace sgb;

struct sgb_ctx {
    int device = 0;
    cudaStream_t stream = nullptr;
    bool owns_stream = false;
    int sm_count = 0;
    uint32_t* status_dev = nullptr;   // 4 words
    uint32_t* status_host = nullptr;  // pinned mirror
    cudaEvent_t sync_event = nullptr;
    bool recording = false;
    std::vector<sgb_buffer*> recording_refs;
    uint64_t recording_launches = 0;
    uint64_t launches = 0;
    // Buffers and timers keep their context alive: sgb_ctx_destroy only drops the caller's reference
    // (the reference's Arc<DeviceCtx>, crates/sg-gpu/src/buffer.rs:229-252).
    std::atomic<int> refs{1};
};

static void ctx_release(sgb_ctx* c)
{
    if (!c) return;
    if (c->refs.fetch_sub(1) != 1) return;
    cudaSetDevice(c->device);
    if (c->stream) cudaStreamSynchronize(c->stream);
    if (c->status_dev) cudaFree(c->status_dev);
    if (c->status_host) cudaFreeHost(c->status_host);
    if (c->sync_event) cudaEventDestroy(c->sync_event);
    if (c->owns_stream && c->stream) cudaStreamDestroy(c->stream);
    delete c;
}


struct sgb_buffer {
    sgb_ctx* ctx;
    void* base;      // allocation (owner only)
    void* ptr;       // this view
    size_t bytes;
    bool owned;      // base came from cudaMalloc
    sgb_buffer* parent;
    std::atomic<int> refs;
};

struct sgb_kernel {
    const KernelEntry* e;
};

// One static handle per registry entry: sgb_kernel_get hands these out, nothing to free.
static const sgb_kernel* kernel_handles(int* count)
{
    static std::vector<sgb_kernel> handles;
    static std::once_flag once;
    std::call_once(once, [] {
        int n = 0;
        const KernelEntry* r = registry(&n);
        handles.resize(n);
        for (int i = 0; i < n; i++) handles[i].e = &r[i];
    });
    *count = (int)handles.size();
    return handles.data();
}

__global__ void step_write_kernel(uint32_t* step, uint32_t pos, uint32_t kv_len_sliding, uint32_t kv_len_global, uint32_t q0)
{
    step[0] = pos;
    step[1] = kv_len_sliding;
    step[2] = kv_len_global;
    step[3] = q0;
}

struct sgb_graph {
    cudaGraph_t graph = nullptr;
    cudaGraphExec_t exec = nullptr;
    std::vector<sgb_buffer*> refs;
    uint64_t launches = 0;
};

struct sgb_timer {
    sgb_ctx* ctx;
    std::vector<cudaEvent_t> ev;
};

#define CUDA_TRY(expr, what)                                                                      \
    do {                                                                                          \
        cudaError_t e__ = (expr);                                                                 \
        if (e__ != cudaSuccess) return set_error(SGB_ERR_CUDA, std::string(what) + ": " + cudaGetErrorString(e__)); \
    } while (0)

extern "C" {

const char* sgb_version(void) { return "sgattn 0.1 (sm_100a)"; }
const char* sgb_last_error(void) { return g_last_error.c_str(); }

static int ctx_create_impl(int device, void* stream, bool make_stream, sgb_ctx** out)
{
    if (!out) return set_error(SGB_ERR_VALIDATION, "sgb_ctx_create: out is NULL");
    *out = nullptr;
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess || n == 0) {
        cudaGetLastError();
        return set_error(SGB_ERR_NO_DEVICE, std::string("no usable CUDA device: ") +
                                                (e != cudaSuccess ? cudaGetErrorString(e) : "device count is 0"));
    }
    if (device < 0 || device >= n) return set_error(SGB_ERR_NO_DEVICE, "device index out of range");
    CUDA_TRY(cudaSetDevice(device), "cudaSetDevice");
    cudaDeviceProp prop;
    CUDA_TRY(cudaGetDeviceProperties(&prop, device), "cudaGetDeviceProperties");
    if (prop.major != 10) {
        char buf[160];
        snprintf(buf, sizeof buf, "device %d is sm_%d%d; this library is built for sm_100a (B200) only", device, prop.major,
                 prop.minor);
        return set_error(SGB_ERR_NO_DEVICE, buf);
    }
    sgb_ctx* c = new sgb_ctx();
    c->device = device;
    c->sm_count = prop.multiProcessorCount;
    if (!make_stream) {
        c->stream = (cudaStream_t)stream;  // NULL is the legacy default stream
    } else {
        e = cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking);
        c->owns_stream = true;
    }
    if (e == cudaSuccess) e = cudaMalloc(&c->status_dev, 16);
    if (e == cudaSuccess) e = cudaMemset(c->status_dev, 0, 16);
    if (e == cudaSuccess) e = cudaMallocHost(&c->status_host, 16);
    if (e == cudaSuccess) e = cudaEventCreateWithFlags(&c->sync_event, cudaEventDisableTiming);
    if (e != cudaSuccess) {
        std::string msg = std::string("context set-up: ") + cudaGetErrorString(e);
        sgb_ctx_destroy(c);
        return set_error(SGB_ERR_CUDA, msg);
    }
    *out = c;
    return SGB_OK;
}

int sgb_ctx_create(int device, sgb_ctx** out) { return ctx_create_impl(device, nullptr, true, out); }
int sgb_ctx_create_on_stream(int device, void* stream, sgb_ctx** out) { return ctx_create_impl(device, stream, false, out); }

void sgb_ctx_destroy(sgb_ctx* c) { ctx_release(c); }

int sgb_ctx_device(const sgb_ctx* c) { return c ? c->device : -1; }
void* sgb_ctx_stream(const sgb_ctx* c) { return c ? (void*)c->stream : nullptr; }
int sgb_ctx_sm_count(const sgb_ctx* c) { return c ? c->sm_count : 0; }
uint64_t sgb_launch_count(const sgb_ctx* c) { return c ? c->launches : 0; }

uint32_t sgb_decode_paged_splits_hint(const sgb_ctx* c, uint32_t n_kv_heads, uint32_t kv_len)
{
    // attn_decode_paged_q8kv_d128 runs 4 warps per CTA and 16 warps per SM.  Two warps per (kv head, split) measured
    // best; the hint makes n_kv_heads * n_splits * 2 warps fill every SM's 16 places exactly (148 SMs, 16 kv heads:
    // 74), and keeps at least 512 tokens per split: below that the launcher's extra sub-splits per split serve a short
    // sequence better than more partials for the combine (16K tokens: 22.5 us per step at 32 splits, 23.4 at 64;
    // 8K: 15.4 at 16, 16.3 at 32).
    const uint32_t sms = c && c->sm_count > 0 ? (uint32_t)c->sm_count : 148u;
    if (n_kv_heads == 0) return 1;
    uint32_t n = sms * 16u / (n_kv_heads * 2u);
    const uint32_t by_len = kv_len / 512u;
    if (n > by_len) n = by_len;
    if (n > 1024u) n = 1024u;
    return n ? n : 1u;
}

int sgb_sync(sgb_ctx* c, uint32_t timeout_ms)
{
    if (!c) return set_error(SGB_ERR_VALIDATION, "sgb_sync: ctx is NULL");
    if (c->recording) return set_error(SGB_ERR_STATE, "sgb_sync while recording a graph");
    if (timeout_ms == 0) timeout_ms = 30000;
    CUDA_TRY(cudaSetDevice(c->device), "cudaSetDevice");
    CUDA_TRY(cudaMemcpyAsync(c->status_host, c->status_dev, 16, cudaMemcpyDeviceToHost, c->stream), "status read");
    CUDA_TRY(cudaEventRecord(c->sync_event, c->stream), "cudaEventRecord");
    const auto t0 = std::chrono::steady_clock::now();
    for (;;) {
        cudaError_t e = cudaEventQuery(c->sync_event);
        if (e == cudaSuccess) break;
        if (e != cudaErrorNotReady) return set_error(SGB_ERR_CUDA, std::string("while waiting: ") + cudaGetErrorString(e));
        const auto ms = std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - t0).count();
        if (ms > (long long)timeout_ms) return set_error(SGB_ERR_TIMEOUT, "sgb_sync: the stream did not drain within the timeout");
        if (ms > 2) std::this_thread::sleep_for(std::chrono::microseconds(50));
    }
    if (c->status_host[0] != 0) {
        char buf[200];
        const uint32_t code = c->status_host[0];
        snprintf(buf, sizeof buf, "a kernel reported %s at site %u (detail %u, %u)",
                 code == 5 ? "a wait that ran out" : code == 6 ? "an out-of-range index" : "an error", c->status_host[1],
                 c->status_host[2], c->status_host[3]);
        cudaMemsetAsync(c->status_dev, 0, 16, c->stream);
        return set_error(code == 5 ? SGB_ERR_TIMEOUT : code == 6 ? SGB_ERR_BOUNDS : SGB_ERR_CUDA, buf);
    }
    return SGB_OK;
}

// ---- buffers ---------------------------------------------------------------------------------------
static sgb_buffer* new_view(sgb_ctx* c, void* base, void* ptr, size_t bytes, bool owned, sgb_buffer* parent)
{
    sgb_buffer* b = new sgb_buffer{c, base, ptr, bytes, owned, parent, {1}};
    if (parent) sgb_buffer_retain(parent);
    c->refs.fetch_add(1);
    return b;
}

int sgb_buffer_create(sgb_ctx* c, size_t bytes, sgb_buffer** out)
{
    if (!c || !out) return set_error(SGB_ERR_VALIDATION, "sgb_buffer_create: NULL argument");
    if (c->recording) return set_error(SGB_ERR_STATE, "sgb_buffer_create while recording a graph");
    CUDA_TRY(cudaSetDevice(c->device), "cudaSetDevice");
    void* p = nullptr;
    const size_t alloc = bytes ? bytes : 16;
    CUDA_TRY(cudaMalloc(&p, alloc), "cudaMalloc");
    cudaError_t e = cudaMemsetAsync(p, 0, alloc, c->stream);
    if (e != cudaSuccess) {
        cudaFree(p);
        return set_error(SGB_ERR_CUDA, std::string("cudaMemsetAsync: ") + cudaGetErrorString(e));
    }
    *out = new_view(c, p, p, bytes, true, nullptr);
    return SGB_OK;
}

int sgb_buffer_adopt(sgb_ctx* c, void* device_ptr, size_t bytes, sgb_buffer** out)
{
    if (!c || !out || !device_ptr) return set_error(SGB_ERR_VALIDATION, "sgb_buffer_adopt: NULL argument");
    *out = new_view(c, nullptr, device_ptr, bytes, false, nullptr);
    return SGB_OK;
}

int sgb_buffer_slice(sgb_buffer* parent, size_t offset, size_t bytes, sgb_buffer** out)
{
    if (!parent || !out) return set_error(SGB_ERR_VALIDATION, "sgb_buffer_slice: NULL argument");
    if (offset > parent->bytes || bytes > parent->bytes - offset)
        return set_error(SGB_ERR_VALIDATION, "sgb_buffer_slice: range outside the parent buffer");
    if (offset % 16) return set_error(SGB_ERR_VALIDATION, "sgb_buffer_slice: offset must be a multiple of 16 bytes");
    *out = new_view(parent->ctx, nullptr, (char*)parent->ptr + offset, bytes, false, parent);
    return SGB_OK;
}

void sgb_buffer_retain(sgb_buffer* b)
{
    if (b) b->refs.fetch_add(1);
}

void sgb_buffer_release(sgb_buffer* b)
{
    if (!b) return;
    if (b->refs.fetch_sub(1) != 1) return;
    if (b->owned && b->base) {
        cudaSetDevice(b->ctx->device);
        cudaStreamSynchronize(b->ctx->stream);
        cudaFree(b->base);
    }
    sgb_buffer* parent = b->parent;
    sgb_ctx* c = b->ctx;
    delete b;
    if (parent) sgb_buffer_release(parent);
    ctx_release(c);
}

void* sgb_buffer_device_ptr(const sgb_buffer* b) { return b ? b->ptr : nullptr; }
size_t sgb_buffer_bytes(const sgb_buffer* b) { return b ? b->bytes : 0; }

static int copy_impl(sgb_buffer* b, size_t offset, void* host, size_t bytes, bool to_device, bool wait)
{
    if (!b || (!host && bytes)) return set_error(SGB_ERR_VALIDATION, "buffer copy: NULL argument");
    if (offset > b->bytes || bytes > b->bytes - offset) return set_error(SGB_ERR_VALIDATION, "buffer copy: range outside the buffer");
    if (b->ctx->recording) return set_error(SGB_ERR_STATE, "buffer copy while recording a graph");
    if (bytes == 0) return SGB_OK;
    CUDA_TRY(cudaSetDevice(b->ctx->device), "cudaSetDevice");
    if (to_device)
        CUDA_TRY(cudaMemcpyAsync((char*)b->ptr + offset, host, bytes, cudaMemcpyHostToDevice, b->ctx->stream), "upload");
    else
        CUDA_TRY(cudaMemcpyAsync(host, (char*)b->ptr + offset, bytes, cudaMemcpyDeviceToHost, b->ctx->stream), "download");
    if (wait) CUDA_TRY(cudaStreamSynchronize(b->ctx->stream), "cudaStreamSynchronize");
    return SGB_OK;
}

int sgb_buffer_upload(sgb_buffer* b, size_t off, const void* host, size_t bytes) { return copy_impl(b, off, (void*)host, bytes, true, true); }
int sgb_buffer_download(sgb_buffer* b, size_t off, void* host, size_t bytes) { return copy_impl(b, off, host, bytes, false, true); }
int sgb_buffer_upload_async(sgb_buffer* b, size_t off, const void* host, size_t bytes) { return copy_impl(b, off, (void*)host, bytes, true, false); }
int sgb_buffer_download_async(sgb_buffer* b, size_t off, void* host, size_t bytes) { return copy_impl(b, off, host, bytes, false, false); }

int sgb_buffer_fill_zero(sgb_buffer* b)
{
    if (!b) return set_error(SGB_ERR_VALIDATION, "sgb_buffer_fill_zero: NULL buffer");
    if (b->bytes == 0) return SGB_OK;
    CUDA_TRY(cudaSetDevice(b->ctx->device), "cudaSetDevice");
    CUDA_TRY(cudaMemsetAsync(b->ptr, 0, b->bytes, b->ctx->stream), "cudaMemsetAsync");
    return SGB_OK;
}

int sgb_host_alloc(size_t bytes, void** out)
{
    if (!out) return set_error(SGB_ERR_VALIDATION, "sgb_host_alloc: out is NULL");
    CUDA_TRY(cudaMallocHost(out, bytes ? bytes : 16), "cudaMallocHost");
    return SGB_OK;
}

void sgb_host_free(void* p)
{
    if (p) cudaFreeHost(p);
}

int sgb_step_write(sgb_buffer* step, uint32_t pos, uint32_t kv_len_sliding, uint32_t kv_len_global, uint32_t q0)
{
    if (!step || step->bytes < 16) return set_error(SGB_ERR_VALIDATION, "sgb_step_write: the step buffer holds 4 x u32");
    if (step->ctx->recording) return set_error(SGB_ERR_STATE, "sgb_step_write while recording: the step buffer is per-replay state");
    // The four words travel as kernel arguments: stream-ordered after every launch queued before
    // it, and no host memory has to outlive the call.
    CUDA_TRY(cudaSetDevice(step->ctx->device), "cudaSetDevice");
    step_write_kernel<<<1, 1, 0, step->ctx->stream>>>((uint32_t*)step->ptr, pos, kv_len_sliding, kv_len_global, q0);
    CUDA_TRY(cudaGetLastError(), "step write");
    step->ctx->launches++;
    return SGB_OK;
}

// ---- registry ---------------------------------------------------------------------------------------
int sgb_kernel_count(void)
{
    int n = 0;
    registry(&n);
    return n;
}

static void fill_info(const KernelEntry* e, sgb_kernel_info* out)
{
    out->name = e->name;
    memcpy(out->workgroup, e->workgroup, sizeof out->workgroup);
    out->bindings = e->bindings;
    out->push_bytes = e->push_bytes;
    out->signature = e->signature;
}

int sgb_kernel_info_at(int index, sgb_kernel_info* out)
{
    int n = 0;
    const KernelEntry* r = registry(&n);
    if (!out || index < 0 || index >= n) return set_error(SGB_ERR_VALIDATION, "sgb_kernel_info_at: index out of range");
    fill_info(&r[index], out);
    return SGB_OK;
}

int sgb_kernel_get(sgb_ctx* c, const char* name, sgb_kernel** out)
{
    if (!c || !name || !out) return set_error(SGB_ERR_VALIDATION, "sgb_kernel_get: NULL argument");
    int n = 0;
    const sgb_kernel* h = kernel_handles(&n);
    for (int i = 0; i < n; i++)
        if (strcmp(h[i].e->name, name) == 0) {
            *out = const_cast<sgb_kernel*>(&h[i]);
            return SGB_OK;
        }
    *out = nullptr;
    return set_error(SGB_ERR_UNKNOWN_KERNEL, std::string("unknown kernel `") + name + "`");
}

int sgb_kernel_describe(const sgb_kernel* k, sgb_kernel_info* out)
{
    if (!k || !out) return set_error(SGB_ERR_VALIDATION, "sgb_kernel_describe: NULL argument");
    fill_info(k->e, out);
    return SGB_OK;
}

// ---- dispatch ---------------------------------------------------------------------------------------
int sgb_dispatch(sgb_ctx* c, const sgb_kernel* k, const sgb_binding* bindings, uint32_t n_bindings, const void* push,
                 size_t push_bytes, const uint32_t groups[3])
{
    if (!c || !k || !groups || (!bindings && n_bindings)) return set_error(SGB_ERR_VALIDATION, "sgb_dispatch: NULL argument");
    const KernelEntry* e = k->e;
    if (n_bindings != e->bindings) {
        char buf[160];
        snprintf(buf, sizeof buf, "%s takes %u bindings, %u given", e->name, e->bindings, n_bindings);
        return set_error(SGB_ERR_VALIDATION, buf);
    }
    if (push_bytes != e->push_bytes || (push_bytes && !push)) {
        char buf[160];
        snprintf(buf, sizeof buf, "%s takes %u push-constant bytes, %zu given", e->name, e->push_bytes, push_bytes);
        return set_error(SGB_ERR_VALIDATION, buf);
    }
    BufView views[16] = {};
    sgb_buffer* bufs[16] = {};
    for (uint32_t i = 0; i < n_bindings; i++) {
        const uint32_t idx = bindings[i].index;
        if (idx >= n_bindings || !bindings[i].buffer || bufs[idx]) {
            char buf[160];
            snprintf(buf, sizeof buf, "%s: bindings must cover indices 0..%u exactly once with non-NULL buffers", e->name,
                     n_bindings - 1);
            return set_error(SGB_ERR_VALIDATION, buf);
        }
        if (bindings[i].buffer->ctx->device != c->device)
            return set_error(SGB_ERR_VALIDATION, std::string(e->name) + ": buffer belongs to another device");
        bufs[idx] = bindings[i].buffer;
        views[idx] = BufView{bindings[i].buffer->ptr, bindings[i].buffer->bytes};
    }
    CUDA_TRY(cudaSetDevice(c->device), "cudaSetDevice");
    std::string err;
    uint64_t launched = 0;
    LaunchArgs a{c->stream, views, push, {groups[0], groups[1], groups[2]}, c->status_dev, c->sm_count, c->device, &err,
                 &launched};
    const int r = e->fn(a);
    if (r != SGB_OK) return set_error(r, err.empty() ? std::string(e->name) + " failed" : err);
    if (c->recording) {
        c->recording_launches += launched;
        for (uint32_t i = 0; i < n_bindings; i++) {
            sgb_buffer_retain(bufs[i]);
            c->recording_refs.push_back(bufs[i]);
        }
    } else {
        c->launches += launched;
    }
    return SGB_OK;
}

int sgb_dispatch_blocking(sgb_ctx* c, const sgb_kernel* k, const sgb_binding* bindings, uint32_t n_bindings, const void* push,
                          size_t push_bytes, const uint32_t groups[3])
{
    const int r = sgb_dispatch(c, k, bindings, n_bindings, push, push_bytes, groups);
    return r != SGB_OK ? r : sgb_sync(c, 0);
}

// ---- graphs -----------------------------------------------------------------------------------------
int sgb_graph_begin(sgb_ctx* c)
{
    if (!c) return set_error(SGB_ERR_VALIDATION, "sgb_graph_begin: ctx is NULL");
    if (c->recording) return set_error(SGB_ERR_STATE, "sgb_graph_begin: already recording");
    CUDA_TRY(cudaSetDevice(c->device), "cudaSetDevice");
    CUDA_TRY(cudaStreamBeginCapture(c->stream, cudaStreamCaptureModeThreadLocal), "cudaStreamBeginCapture");
    c->recording = true;
    c->recording_launches = 0;
    return SGB_OK;
}

int sgb_graph_end(sgb_ctx* c, sgb_graph** out)
{
    if (!c || !out) return set_error(SGB_ERR_VALIDATION, "sgb_graph_end: NULL argument");
    if (!c->recording) return set_error(SGB_ERR_STATE, "sgb_graph_end without sgb_graph_begin");
    c->recording = false;
    sgb_graph* g = new sgb_graph();
    g->refs.swap(c->recording_refs);
    g->launches = c->recording_launches;
    cudaError_t e = cudaStreamEndCapture(c->stream, &g->graph);
    if (e == cudaSuccess) e = cudaGraphInstantiate(&g->exec, g->graph, 0);
    if (e != cudaSuccess) {
        std::string msg = std::string("graph capture: ") + cudaGetErrorString(e);
        sgb_graph_destroy(g);
        return set_error(SGB_ERR_CUDA, msg);
    }
    *out = g;
    return SGB_OK;
}

int sgb_graph_launch(sgb_ctx* c, sgb_graph* g)
{
    if (!c || !g || !g->exec) return set_error(SGB_ERR_VALIDATION, "sgb_graph_launch: NULL argument");
    if (c->recording) return set_error(SGB_ERR_STATE, "sgb_graph_launch while recording");
    CUDA_TRY(cudaSetDevice(c->device), "cudaSetDevice");
    CUDA_TRY(cudaGraphLaunch(g->exec, c->stream), "cudaGraphLaunch");
    c->launches += g->launches;
    return SGB_OK;
}

void sgb_graph_destroy(sgb_graph* g)
{
    if (!g) return;
    if (g->exec) cudaGraphExecDestroy(g->exec);
    if (g->graph) cudaGraphDestroy(g->graph);
    for (sgb_buffer* b : g->refs) sgb_buffer_release(b);
    delete g;
}

// ---- timers -----------------------------------------------------------------------------------------
int sgb_timer_create(sgb_ctx* c, uint32_t n, sgb_timer** out)
{
    if (!c || !out || n == 0) return set_error(SGB_ERR_VALIDATION, "sgb_timer_create: bad argument");
    CUDA_TRY(cudaSetDevice(c->device), "cudaSetDevice");
    sgb_timer* t = new sgb_timer{c, {}};
    c->refs.fetch_add(1);
    t->ev.resize(n, nullptr);
    for (uint32_t i = 0; i < n; i++) {
        cudaError_t e = cudaEventCreate(&t->ev[i]);
        if (e != cudaSuccess) {
            sgb_timer_destroy(t);
            return set_error(SGB_ERR_CUDA, std::string("cudaEventCreate: ") + cudaGetErrorString(e));
        }
    }
    *out = t;
    return SGB_OK;
}

int sgb_timer_stamp(sgb_ctx* c, sgb_timer* t, uint32_t index)
{
    if (!c || !t || index >= t->ev.size()) return set_error(SGB_ERR_VALIDATION, "sgb_timer_stamp: bad argument");
    CUDA_TRY(cudaSetDevice(c->device), "cudaSetDevice");
    CUDA_TRY(cudaEventRecordWithFlags(t->ev[index], c->stream, c->recording ? cudaEventRecordExternal : cudaEventRecordDefault),
             "cudaEventRecord");
    return SGB_OK;
}

int sgb_timer_read_ns(sgb_timer* t, uint64_t* out_ns, uint32_t n)
{
    if (!t || !out_ns || n > t->ev.size()) return set_error(SGB_ERR_VALIDATION, "sgb_timer_read_ns: bad argument");
    CUDA_TRY(cudaSetDevice(t->ctx->device), "cudaSetDevice");
    for (uint32_t i = 0; i < n; i++) {
        CUDA_TRY(cudaEventSynchronize(t->ev[i]), "cudaEventSynchronize");
        float ms = 0.0f;
        CUDA_TRY(cudaEventElapsedTime(&ms, t->ev[0], t->ev[i]), "cudaEventElapsedTime");
        out_ns[i] = (uint64_t)((double)ms * 1.0e6 + 0.5);
    }
    return SGB_OK;
}

void sgb_timer_destroy(sgb_timer* t)
{
    if (!t) return;
    for (cudaEvent_t e : t->ev)
        if (e) cudaEventDestroy(e);
    sgb_ctx* c = t->ctx;
    delete t;
    ctx_release(c);
}

}  // extern "C"
