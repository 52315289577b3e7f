// sg_gpu.hpp -- header-only C++17 mirror of the slice of super-gemma's `sg-gpu` Rust API that the
// attention path uses, over the C ABI of sgattn.h.  Same names and argument meaning as the
// reference (crates/sg-gpu/src/lib.rs:20-44): GpuContext (context.rs:103), Buffer<T> / BufferBinding
// (buffer.rs:80), Kernel / load_kernel (kernel.rs:79), dispatch / dispatch_blocking (graph.rs:203,
// exec.rs:12), record_graph / submit_blocking (graph.rs:523-528,640), StepState (graph.rs:29-61),
// GpuTimer (graph.rs:404-473).  Errors are the reference's GpuError variants as exceptions.
#pragma once

#include <cstdint>
#include <cstring>
#include <functional>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "sgattn.h"

namespace sg_gpu {

struct GpuError : std::runtime_error {
    int code;
    GpuError(int c, const std::string& m) : std::runtime_error(m), code(c) {}
};
struct NoDevice : GpuError { using GpuError::GpuError; };
struct UnknownKernel : GpuError { using GpuError::GpuError; };
struct Validation : GpuError { using GpuError::GpuError; };

inline void check(int code)
{
    if (code == SGB_OK) return;
    const std::string msg = sgb_last_error();
    switch (code) {
        case SGB_ERR_NO_DEVICE: throw NoDevice(code, msg);
        case SGB_ERR_UNKNOWN_KERNEL: throw UnknownKernel(code, msg);
        case SGB_ERR_VALIDATION: throw Validation(code, msg);
        default: throw GpuError(code, msg);
    }
}

// Per-step dynamic state read by the kernels from the step buffer (graph.rs:29-48).
struct StepState {
    uint32_t pos = 0, kv_len_sliding = 0, kv_len_global = 0, q0 = 0;
};
constexpr uint64_t STEP_WORDS = 4;

class GpuContext;

// A typed view of device memory; copies share the allocation (the reference's Arc).
template <class T>
class Buffer {
public:
    Buffer() = default;
    Buffer(const Buffer& o) : h_(o.h_) { sgb_buffer_retain(h_); }
    Buffer(Buffer&& o) noexcept : h_(std::exchange(o.h_, nullptr)) {}
    Buffer& operator=(Buffer o) noexcept { std::swap(h_, o.h_); return *this; }
    ~Buffer() { sgb_buffer_release(h_); }

    uint64_t len() const { return sgb_buffer_bytes(h_) / sizeof(T); }
    // Buffer::slice (buffer.rs:112-124): element range sharing the allocation.
    Buffer slice(uint64_t start, uint64_t stop) const
    {
        sgb_buffer* out = nullptr;
        check(sgb_buffer_slice(h_, start * sizeof(T), (stop - start) * sizeof(T), &out));
        return Buffer(out);
    }
    std::vector<T> read() const
    {
        std::vector<T> v(len());
        check(sgb_buffer_download(h_, 0, v.data(), v.size() * sizeof(T)));
        return v;
    }
    void write(const std::vector<T>& v) { check(sgb_buffer_upload(h_, 0, v.data(), v.size() * sizeof(T))); }
    sgb_buffer* raw() const { return h_; }

private:
    friend class GpuContext;
    explicit Buffer(sgb_buffer* h) : h_(h) {}
    sgb_buffer* h_ = nullptr;
};

struct BufferBinding {
    uint32_t index;
    sgb_buffer* buf;
    template <class T>
    static BufferBinding buffer(uint32_t index, const Buffer<T>& b) { return {index, b.raw()}; }
};

struct Kernel {
    sgb_kernel* raw = nullptr;
    std::string name;
    uint32_t workgroup[3] = {1, 1, 1};
    // Workgroup count covering n invocations on x (kernel.rs:56-58).
    std::vector<uint32_t> groups_for(uint64_t n) const { return {uint32_t((n + workgroup[0] - 1) / workgroup[0]), 1, 1}; }
};

class CommandGraph {
public:
    explicit CommandGraph(sgb_graph* g) : g_(g) {}
    CommandGraph(CommandGraph&& o) noexcept : g_(std::exchange(o.g_, nullptr)) {}
    CommandGraph(const CommandGraph&) = delete;
    ~CommandGraph() { sgb_graph_destroy(g_); }
    sgb_graph* raw() const { return g_; }

private:
    sgb_graph* g_;
};

class GpuContext {
public:
    explicit GpuContext(int device = 0) { check(sgb_ctx_create(device, &c_)); }
    GpuContext(const GpuContext&) = delete;
    ~GpuContext() { sgb_ctx_destroy(c_); }

    template <class T>
    Buffer<T> new_buffer(uint64_t len)  // zero-initialised (buffer.rs:257-275)
    {
        sgb_buffer* b = nullptr;
        check(sgb_buffer_create(c_, len * sizeof(T), &b));
        return Buffer<T>(b);
    }
    template <class T>
    Buffer<T> buffer_from_iter(const std::vector<T>& data)  // buffer.rs:278
    {
        Buffer<T> b = new_buffer<T>(data.size());
        b.write(data);
        return b;
    }
    Buffer<uint32_t> new_step_buffer() { return new_buffer<uint32_t>(STEP_WORDS); }
    void write_step(const StepState& s, const Buffer<uint32_t>& buf)  // StepState::write_to
    {
        check(sgb_step_write(buf.raw(), s.pos, s.kv_len_sliding, s.kv_len_global, s.q0));
    }

    Kernel load_kernel(const std::string& name)  // kernel.rs:79
    {
        Kernel k;
        check(sgb_kernel_get(c_, name.c_str(), &k.raw));
        sgb_kernel_info info;
        check(sgb_kernel_describe(k.raw, &info));
        k.name = info.name;
        std::memcpy(k.workgroup, info.workgroup, sizeof k.workgroup);
        return k;
    }

    // GraphRecorder::dispatch (graph.rs:203-211): push is a POD block or nullptr.
    template <class P>
    void dispatch(const Kernel& k, const std::vector<BufferBinding>& bindings, const P* push, const std::vector<uint32_t>& groups)
    {
        submit_(sgb_dispatch, k, bindings, push, push ? sizeof(P) : 0, groups);
    }
    template <class P>
    void dispatch_blocking(const Kernel& k, const std::vector<BufferBinding>& bindings, const P* push,
                           const std::vector<uint32_t>& groups)  // exec.rs:12-23
    {
        submit_(sgb_dispatch_blocking, k, bindings, push, push ? sizeof(P) : 0, groups);
    }
    void sync(uint32_t timeout_ms = 0) { check(sgb_sync(c_, timeout_ms)); }

    // record_graph (graph.rs:523-528): dispatches made inside `record` are captured, not run.
    CommandGraph record_graph(const std::function<void(GpuContext&)>& record)
    {
        check(sgb_graph_begin(c_));
        sgb_graph* g = nullptr;
        try {
            record(*this);
        } catch (...) {
            if (sgb_graph_end(c_, &g) == SGB_OK) sgb_graph_destroy(g);
            throw;
        }
        check(sgb_graph_end(c_, &g));
        return CommandGraph(g);
    }
    void submit_blocking(const CommandGraph& g, uint32_t timeout_ms = 0)  // graph.rs:640-642, finite wait
    {
        check(sgb_graph_launch(c_, g.raw()));
        sync(timeout_ms);
    }
    sgb_ctx* raw() const { return c_; }

private:
    template <class F>
    void submit_(F fn, const Kernel& k, const std::vector<BufferBinding>& bindings, const void* push, size_t push_bytes,
                 const std::vector<uint32_t>& groups)
    {
        std::vector<sgb_binding> raw;
        for (const BufferBinding& b : bindings) raw.push_back({b.index, b.buf});
        uint32_t g[3] = {1, 1, 1};
        for (size_t i = 0; i < groups.size() && i < 3; i++) g[i] = groups[i];
        check(fn(c_, k.raw, raw.data(), uint32_t(raw.size()), push, push_bytes, g));
    }
    sgb_ctx* c_ = nullptr;
};

// GpuTimer (graph.rs:404-473): stamps recorded on the context's stream, read back in nanoseconds.
class GpuTimer {
public:
    GpuTimer(GpuContext& ctx, uint32_t n) : ctx_(ctx.raw()), n_(n) { check(sgb_timer_create(ctx_, n, &t_)); }
    GpuTimer(const GpuTimer&) = delete;
    ~GpuTimer() { sgb_timer_destroy(t_); }
    void stamp(uint32_t i) { check(sgb_timer_stamp(ctx_, t_, i)); }
    std::vector<uint64_t> read_ns()
    {
        std::vector<uint64_t> v(n_);
        check(sgb_timer_read_ns(t_, v.data(), n_));
        return v;
    }

private:
    sgb_ctx* ctx_;
    sgb_timer* t_ = nullptr;
    uint32_t n_;
};

// Page tables for the paged kernels: the radix trie of docs/plans/04-kv-cache.md:40-51 at page granularity
// over a pool of physical pages (constants crates/sg-cache/src/lib.rs:9-13).  Host side only.
class PageCache {
public:
    struct Sequence {
        uint64_t handle = 0;
        std::vector<uint32_t> table;  // logical page -> physical page
        uint64_t reused_tokens = 0;   // K/V of this many leading tokens is already in the pool
    };
    static constexpr uint32_t MIN_PAGE_SIZE = 16, MAX_PAGE_SIZE = 512, DEFAULT_PAGE_SIZE = 256;

    explicit PageCache(uint32_t pool_pages, uint32_t page_tokens = DEFAULT_PAGE_SIZE) : page_(page_tokens)
    {
        check(sgb_cache2_create(page_tokens, pool_pages, &c_));
    }
    PageCache(const PageCache&) = delete;
    ~PageCache() { sgb_cache2_destroy(c_); }

    uint64_t lookup(const std::vector<int32_t>& tokens)
    {
        uint64_t matched = 0;
        check(sgb_cache2_lookup(c_, tokens.data(), tokens.size(), &matched));
        return matched;
    }
    Sequence acquire(const std::vector<int32_t>& tokens, uint64_t capacity_tokens = 0)
    {
        const uint64_t cap = capacity_tokens > tokens.size() ? capacity_tokens : tokens.size();
        Sequence s;
        s.table.resize(size_t((cap + page_ - 1) / page_) + 1);
        uint32_t n_pages = 0;
        check(sgb_cache2_acquire(c_, tokens.data(), tokens.size(), cap, s.table.data(), uint32_t(s.table.size()), &n_pages,
                                 &s.reused_tokens, &s.handle));
        s.table.resize(n_pages);
        return s;
    }
    void commit(const Sequence& s, const std::vector<int32_t>& tokens) { check(sgb_cache2_commit(c_, s.handle, tokens.data(), tokens.size())); }
    void release(const Sequence& s) { check(sgb_cache2_release(c_, s.handle)); }
    sgb_cache2_stats_t stats() const
    {
        sgb_cache2_stats_t st;
        check(sgb_cache2_stats(c_, &st));
        return st;
    }

private:
    sgb_cache2* c_ = nullptr;
    uint32_t page_;
};

}  // namespace sg_gpu
