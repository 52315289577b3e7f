// A C++ caller of the library through include/sg_gpu.hpp, written the way the reference's own kernel
// test is (crates/sg-gpu/tests/parity_attn.rs:61-155, attn_decode_sliding_matches_reference): same
// generator, same seed, same cases, same tolerance; the f64 oracle is oracle/sg_oracle.c, linked in
// as the checker.  Exit code 0 = all cases pass, 77 = no usable GPU (the reference's tests skip too).
#include <cmath>
#include <cstdio>
#include <vector>

#include "sg_gpu.hpp"

extern "C" {
void sgo_rng_seed(uint64_t* state, uint64_t seed);
void sgo_rng_f32_vec(uint64_t* state, float* out, size_t n);
void sgo_through_f16(const float* x, float* out, size_t n);
void sgo_f32_to_f16_vec(const float* x, uint16_t* out, size_t n);
void sgo_f16_to_f32_vec(const uint16_t* x, float* out, size_t n);
void sgo_attention_head(const float* q, const float* k, const float* v, size_t i, int qh, int n_q, int n_kv, int hd, double scale,
                        size_t t0, size_t t1, float* out);
}

using namespace sg_gpu;

constexpr int N_Q_HEADS = 32, SL_KV_HEADS = 16, SL_DIM = 256, SL_PART_STRIDE = SL_DIM + 2;
constexpr float SL_SCALE = 0.0625f, ATOL = 1e-2f, RTOL = 1e-2f;

struct PushSplitScale {
    uint32_t n_splits;
    float scale;
};

static std::vector<float> f16_vec(uint64_t* rng, size_t n)
{
    std::vector<float> x(n), y(n);
    sgo_rng_f32_vec(rng, x.data(), n);
    sgo_through_f16(x.data(), y.data(), n);
    return y;
}
static std::vector<uint16_t> bits(const std::vector<float>& x)
{
    std::vector<uint16_t> b(x.size());
    sgo_f32_to_f16_vec(x.data(), b.data(), x.size());
    return b;
}

int main()
{
    try {
        GpuContext ctx(0);
        Kernel part_k = ctx.load_kernel("attn_decode_sliding");
        Kernel red_k = ctx.load_kernel("attn_reduce_d256");
        uint64_t rng;
        sgo_rng_seed(&rng, 0xA77);
        const std::pair<size_t, uint32_t> cases[] = {{17, 1}, {17, 4}, {1024, 8}};
        for (auto [kv_len, n_splits] : cases) {
            auto q = f16_vec(&rng, N_Q_HEADS * SL_DIM);
            auto k = f16_vec(&rng, kv_len * SL_KV_HEADS * SL_DIM);
            auto v = f16_vec(&rng, kv_len * SL_KV_HEADS * SL_DIM);
            auto q_buf = ctx.buffer_from_iter(bits(q)), k_buf = ctx.buffer_from_iter(bits(k)), v_buf = ctx.buffer_from_iter(bits(v));
            auto part_buf = ctx.new_buffer<float>(uint64_t(N_Q_HEADS) * n_splits * SL_PART_STRIDE);
            auto out_buf = ctx.new_buffer<uint16_t>(N_Q_HEADS * SL_DIM);
            auto step = ctx.new_step_buffer();
            StepState st;
            st.kv_len_sliding = uint32_t(kv_len);
            ctx.write_step(st, step);
            const PushSplitScale push{n_splits, SL_SCALE};
            ctx.dispatch_blocking(part_k,
                                  {BufferBinding::buffer(0, q_buf), BufferBinding::buffer(1, k_buf), BufferBinding::buffer(2, v_buf),
                                   BufferBinding::buffer(3, part_buf), BufferBinding::buffer(4, step)},
                                  &push, {SL_KV_HEADS, n_splits, 1});
            ctx.dispatch_blocking(red_k, {BufferBinding::buffer(0, part_buf), BufferBinding::buffer(1, out_buf)}, &n_splits,
                                  {N_Q_HEADS, 1, 1});
            const auto out_bits = out_buf.read();
            std::vector<float> got(out_bits.size()), want(SL_DIM);
            sgo_f16_to_f32_vec(out_bits.data(), got.data(), got.size());
            for (int qh = 0; qh < N_Q_HEADS; qh++) {
                sgo_attention_head(q.data(), k.data(), v.data(), 0, qh, N_Q_HEADS, SL_KV_HEADS, SL_DIM, SL_SCALE, 0, kv_len - 1,
                                   want.data());
                for (int d = 0; d < SL_DIM; d++) {
                    const float g = got[qh * SL_DIM + d], w = want[d];
                    if (!(std::fabs(g - w) - RTOL * std::fabs(w) <= ATOL)) {
                        std::printf("decode_sliding kv_len=%zu splits=%u qh=%d d=%d: got %g want %g\n", kv_len, n_splits, qh, d, g, w);
                        return 1;
                    }
                }
            }
        }
        bool unknown = false;
        try {
            ctx.load_kernel("no_such_kernel");
        } catch (const UnknownKernel&) {
            unknown = true;
        }
        if (!unknown) return 2;
        std::printf("parity_decode_sliding: ok\n");
        return 0;
    } catch (const NoDevice& e) {
        std::printf("skipping: no usable GPU (%s)\n", e.what());
        return 77;
    } catch (const GpuError& e) {
        std::printf("GpuError %d: %s\n", e.code, e.what());
        return 3;
    }
}
