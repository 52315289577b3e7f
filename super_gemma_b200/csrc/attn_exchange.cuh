// The exchange of one merged row between the ranks of a sequence-parallel decode, as a device function:
// used by attn_reduce_exchange_d128 (one CTA per row) and by the decode kernel that folds the combine and
// the exchange into its own tail.  A GROUP of 64 threads (two whole warps) holds the row's locally merged
// (acc, m, l), two dims per thread, and
//   1. stores it into slot [parity][rank][row] of EVERY rank's exchange buffer with plain peer stores over
//      NVLink, fences, then release-stores the row's epoch into that slot's flag on every rank;
//   2. acquire-polls the local flags of all ranks for this row (bounded; DEV_ERR_TIMEOUT after the limit);
//   3. merges the ranks' rows in rank order (merge_splits_running) and writes out = acc / l.
// Exchange buffer of one rank, in 4-byte words: data f32[2][world][rows][130], flags u32[2][world][rows],
// epoch u32[rows]; zeroed once before first use, after all ranks have allocated theirs.  Slots alternate with
// the parity of the per-row epoch: a rank can be at most one step ahead of a peer that still reads the other
// parity, because its next step needs that peer's row of the current one.  After a timeout the row is NaN
// and the row's epoch is NOT advanced: the next launch on this buffer fails fast on the same flag instead of
// overwriting a slot that a slow peer may still read; the host must then re-zero every rank's buffer under
// a barrier before using it again.  No multimem, no TMA: plain ld/st.
#pragma once

#include "attn_merge.cuh"
#include "sgb_common.cuh"

namespace sgb {

constexpr int XCHG_HD = 128;
constexpr int XCHG_ROWF = XCHG_HD + 2;

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v)
{
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p)
{
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__host__ __device__ inline size_t xchg_words(size_t world, size_t rows) { return 2 * world * rows * XCHG_ROWF + 2 * world * rows + rows; }

// t = 0..63 is the thread's index in its group, bar_id a named barrier no other group of the CTA uses,
// timed_out a shared-memory word of the group that is zero on entry.  t_phase (thread 0 of the group, may be
// nullptr) receives the global timer after step 1 and after step 2.
__device__ __forceinline__ void exchange_row(const float (&acc_in)[2], MergeState st_in, size_t row, size_t rows, int t, uint32_t bar_id,
                                             uint32_t* timed_out, float* xbuf, const unsigned long long* __restrict__ peers,
                                             uint32_t world, uint32_t rank, long long wait_cycles, uint32_t* status,
                                             float* __restrict__ out, unsigned long long* t_phase)
{
    constexpr int HD = XCHG_HD, ROWF = XCHG_ROWF;
    const int d0 = 2 * t;
    const size_t flags_off = 2 * (size_t)world * rows * ROWF, epoch_off = flags_off + 2 * (size_t)world * rows;
    uint32_t* my_words = reinterpret_cast<uint32_t*>(xbuf);
    const uint32_t epoch = __ldcg(my_words + epoch_off + row) + 1;  // written only by this row's group of the previous launch
    const uint32_t parity = epoch & 1;
    const size_t slot = ((size_t)parity * world + rank) * rows + row;
    for (uint32_t p = 0; p < world; p++) {
        float* dst = reinterpret_cast<float*>(peers[p]) + slot * ROWF;
        *reinterpret_cast<float2*>(dst + d0) = make_float2(acc_in[0], acc_in[1]);
        if (t == 0) *reinterpret_cast<float2*>(dst + HD) = make_float2(st_in.m, st_in.l);
    }
    __threadfence_system();
    named_barrier_sync(bar_id, 64);
    if ((uint32_t)t < world) st_release_sys(reinterpret_cast<uint32_t*>(peers[t]) + flags_off + slot, epoch);
    if (t_phase != nullptr && t == 0) t_phase[0] = globaltimer_ns();

    if ((uint32_t)t < world) {
        const uint32_t* flag = my_words + flags_off + ((size_t)parity * world + t) * rows + row;
        const long long limit = wait_cycles > 0 ? wait_cycles : WAIT_LIMIT_CYCLES;
        const long long t0 = clock64();
        while (ld_acquire_sys(flag) != epoch) {
            if (clock64() - t0 > limit) {
                *timed_out = 1;
                report_error(status, DEV_ERR_TIMEOUT, 601, (uint32_t)row, (uint32_t)t);
                break;
            }
            __nanosleep(100);
        }
    }
    named_barrier_sync(bar_id, 64);
    if (t_phase != nullptr && t == 0) t_phase[1] = globaltimer_ns();

    float acc[2];
    const MergeState st = merge_splits_running<HD, 2>(xbuf + ((size_t)parity * world * rows + row) * ROWF, rows * ROWF, world, d0, acc);
    const bool bad = *reinterpret_cast<volatile uint32_t*>(timed_out) != 0;
    const float nan = __int_as_float(0x7fc00000);  // a row that gave up is NaN, never stale data
    *reinterpret_cast<float2*>(out + row * HD + d0) = bad ? make_float2(nan, nan) : make_float2(acc[0] / st.l, acc[1] / st.l);
    if (t == 0 && !bad) my_words[epoch_off + row] = epoch;
}

}  // namespace sgb
