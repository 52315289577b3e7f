// The split-K combine, stated once: every kernel that merges (acc, m, l) partials -- the stand-alone
// attn_reduce_* kernels, the allocation-free decode entry point and the exchange between ranks -- walks
// the partials in ascending index order with a running maximum, exactly as attn_reduce.wgsl:40-52 does:
//     m_new = max(m, m_s);  ca = exp(m - m_new);  cb = exp(m_s - m_new)
//     acc = acc * ca + acc_s * cb;  l = l * ca + l_s * cb;  m = m_new
// so all of them produce the same bits from the same partials, and reruns are bit-identical.
// The loads of 32 splits are issued before the dependent arithmetic on them, so the chain costs one
// memory latency per 32 splits, not one per split.
#pragma once

#include "sgb_common.cuh"

namespace sgb {

struct MergeState {
    float m, l;
};

// All 32 lanes of a warp call this for the SAME row; a lane merges N consecutive dims starting at d0
// (N = 1 or 2: partial rows are 8-byte, not 16-byte, aligned).  `row_base` points at split 0 of the row,
// consecutive splits are `s_stride` floats apart, a partial is acc[HD], m, l.  Lane u fetches (m, l) of
// split s0 + u for the whole warp.  The partials may have been written by other CTAs of the same grid or
// by another GPU: they are read through L2 (ld.cg), never from this SM's L1.
template <int HD, int N>
__device__ __forceinline__ MergeState merge_splits_running(const float* row_base, size_t s_stride, uint32_t n_splits, int d0,
                                                           float (&acc)[N])
{
    static_assert(N == 1 || N == 2, "a lane owns 1 or 2 dims");
    constexpr int BATCH = 32;
    const uint32_t lane = threadIdx.x & 31u;
    float m = NEG_SENTINEL, l = 0.0f;
#pragma unroll
    for (int d = 0; d < N; d++) acc[d] = 0.0f;
    for (uint32_t s0 = 0; s0 < n_splits; s0 += BATCH) {
        float v[BATCH][N];
        float2 ml = make_float2(NEG_SENTINEL, 0.0f);
        if (s0 + lane < n_splits) ml = __ldcg(reinterpret_cast<const float2*>(row_base + (size_t)(s0 + lane) * s_stride + HD));
#pragma unroll
        for (int u = 0; u < BATCH; u++) {
            if (s0 + u < n_splits) {
                const float* p = row_base + (size_t)(s0 + u) * s_stride + d0;
                if constexpr (N == 2) {
                    const float2 x = __ldcg(reinterpret_cast<const float2*>(p));
                    v[u][0] = x.x, v[u][1] = x.y;
                } else {
                    v[u][0] = __ldcg(p);
                }
            }
        }
#pragma unroll
        for (int u = 0; u < BATCH; u++) {
            const float ms = __shfl_sync(0xffffffffu, ml.x, u), ls = __shfl_sync(0xffffffffu, ml.y, u);
            if (s0 + u < n_splits) {
                const float m_new = fmaxf(m, ms);
                const float ca = __expf(m - m_new), cb = __expf(ms - m_new);  // empty split: exp(-3e38 - m) = 0
#pragma unroll
                for (int d = 0; d < N; d++) acc[d] = fmaf(acc[d], ca, __fmul_rn(v[u][d], cb));  // one spelling, one rounding order
                l = fmaf(l, ca, __fmul_rn(ls, cb));
                m = m_new;
            }
        }
    }
    return MergeState{m, l};
}

}  // namespace sgb
