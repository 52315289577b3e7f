// The split-K combine, stated once: every kernel that merges (acc, m, l) partials -- the stand-alone
// attn_reduce_* kernels, the allocation-free decode entry point and the exchange between ranks -- walks
// the partials in ascending index order with a running maximum, exactly as attn_reduce.wgsl:40-52 does:
//     m_new = max(m, m_s);  ca = exp(m - m_new);  cb = exp(m_s - m_new)
//     acc = acc * ca + acc_s * cb;  l = l * ca + l_s * cb;  m = m_new
// so all of them produce the same bits from the same partials, and reruns are bit-identical.
// The loads of up to NB x 32 splits are issued together, and the part of the recurrence that is the same for every dim of a
// row -- the running maximum and the two factors ca, cb of each split -- is taken out of the per-dim chain: lane u
// owns split s0 + u, the running maximum is a prefix maximum over the lanes (five shuffles), every lane computes its
// split's ca and cb at once, and what remains serial is one fused multiply-add per split and dim.  The values of m, ca,
// cb and the order of the multiply-adds are exactly those of the sequential statement, so the bits are too.
#pragma once

#include "sgb_common.cuh"

namespace sgb {

struct MergeState {
    float m, l;
};

// One batch of up to 32 partials that are already in registers: lane u holds (m, l) of partial u in `ml`, every lane
// holds its N dims of all 32 partials in `v`; partials u >= n_valid do not exist.  Continues the running (m, l, acc).
template <int N>
__device__ __forceinline__ void merge_batch(const float (&v)[32][N], float2 ml, uint32_t n_valid, float& m, float& l, float (&acc)[N])
{
    const uint32_t lane = threadIdx.x & 31u;
    const bool mine = lane < n_valid;
    const float ms = mine ? ml.x : NEG_SENTINEL, ls = mine ? ml.y : 0.0f;  // lanes past the end: an empty partial, skipped below
    float pm = ms;  // inclusive prefix maximum over the lanes, then joined with the maximum carried in
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
        const float t = __shfl_up_sync(0xffffffffu, pm, off);
        if (lane >= (uint32_t)off) pm = fmaxf(pm, t);
    }
    pm = fmaxf(pm, m);                                  // running maximum after this lane's partial
    float prev = __shfl_up_sync(0xffffffffu, pm, 1);    // ... and before it
    if (lane == 0) prev = m;
    const float ca = __expf(prev - pm), cb = __expf(ms - pm);  // empty partial: exp(-3e38 - m) = 0
    const float lcb = __fmul_rn(ls, cb);
#pragma unroll
    for (int u = 0; u < 32; u++) {
        const float a = __shfl_sync(0xffffffffu, ca, u), c = __shfl_sync(0xffffffffu, cb, u), lb = __shfl_sync(0xffffffffu, lcb, u);
        if ((uint32_t)u < n_valid) {
#pragma unroll
            for (int d = 0; d < N; d++) acc[d] = fmaf(acc[d], a, __fmul_rn(v[u][d], c));  // one spelling, one rounding order
            l = fmaf(l, a, lb);
        }
    }
    m = __shfl_sync(0xffffffffu, pm, 31);  // lanes past the end carry the last real maximum along
}

// All 32 lanes of a warp call this for the SAME row; a lane merges N consecutive dims starting at d0
// (N = 1 or 2: partial rows are 8-byte, not 16-byte, aligned).  `row_base` points at split 0 of the row,
// consecutive splits are `s_stride` floats apart, a partial is acc[HD], m, l.  Lane u fetches (m, l) of
// split s0 + u for the whole warp.  The partials may have been written by other CTAs of the same grid or
// by another GPU: they are read through L2 (ld.cg), never from this SM's L1.
template <int HD, int N, int NB = 1>
__device__ __forceinline__ MergeState merge_splits_running(const float* row_base, size_t s_stride, uint32_t n_splits, int d0,
                                                           float (&acc)[N])
{
    static_assert(N == 1 || N == 2, "a lane owns 1 or 2 dims");
    constexpr int BATCH = 32;  // splits per batch: one per lane for the (m, l) pairs
    const uint32_t lane = threadIdx.x & 31u;
    float m = NEG_SENTINEL, l = 0.0f;
#pragma unroll
    for (int d = 0; d < N; d++) acc[d] = 0.0f;
    for (uint32_t s0 = 0; s0 < n_splits; s0 += NB * BATCH) {
        // Straight-line loads of NB batches: indices past the end are clamped to the last split (a valid address) and
        // their values ignored below, so that nothing stands between one load and the next and all of them are in
        // flight together: NB * 32 splits cost one memory latency.
        float v[NB][BATCH][N];
        float2 ml[NB];
#pragma unroll
        for (int b = 0; b < NB; b++) {
            const uint32_t s_mine = min(s0 + b * BATCH + lane, n_splits - 1);
            ml[b] = __ldcg(reinterpret_cast<const float2*>(row_base + (size_t)s_mine * s_stride + HD));
#pragma unroll
            for (int u = 0; u < BATCH; u++) {
                const float* p = row_base + (size_t)min(s0 + (uint32_t)(b * BATCH + u), n_splits - 1) * s_stride + d0;
                if constexpr (N == 2) {
                    const float2 x = __ldcg(reinterpret_cast<const float2*>(p));
                    v[b][u][0] = x.x, v[b][u][1] = x.y;
                } else {
                    v[b][u][0] = __ldcg(p);
                }
            }
        }
#pragma unroll
        for (int b = 0; b < NB; b++) {
            const uint32_t sb = s0 + b * BATCH;
            if (sb >= n_splits) break;
            merge_batch<N>(v[b], ml[b], n_splits - sb, m, l, acc);
        }
    }
    return MergeState{m, l};
}

}  // namespace sgb
